"""Host-memory tier of the prefix cache: blocks evicted from the (tiny) device cache come back from
host memory and the request that reuses them skips their prefill with identical output."""
import torch

from xllm_b200 import LLM, SamplingParams


def test_evicted_prefix_returns_from_host():
    llm = LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=14, max_seqs_per_batch=2,
              max_tokens_per_batch=128, enable_graph=False, enable_prefix_cache=True, host_kv_blocks=64)
    eng = llm.engine
    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, 32000, (100,), generator=g).tolist()
    others = [torch.randint(0, 32000, (120,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    first = llm.generate([a], sp)[0].outputs[0].token_ids
    for o in others:                      # push A's blocks out of the 13-block device cache
        llm.generate([o], sp)
    st = eng.host_tier.stats()
    assert st["saved"] >= 6, st           # A's six full blocks went to the host tier
    bm = eng.scheduler.block_manager(0)
    chain = eng.rt.block_hash_chain(a, 16, 0)
    assert bm.lookup(*chain[0]) < 0       # no longer on the device
    q0 = eng.scheduler.block_stats(0).match_hits_blocks
    again = llm.generate([a], sp)[0].outputs[0].token_ids
    assert again == first
    assert eng.host_tier.stats()["loaded"] >= 6
    assert eng.scheduler.block_stats(0).match_hits_blocks - q0 >= 6   # served as prefix hits


def test_blocks_dropped_by_the_host_tier_come_back_from_the_store(tmp_path):
    """Device cache of 13 blocks, host tier of 4: a 100-token prompt's blocks fall through both into the
    directory store; a second engine (a restarted instance) sharing the directory reuses them."""
    kw = dict(devices="cpu", dtype="float32", block_size=16, num_blocks=14, max_seqs_per_batch=2, max_tokens_per_batch=128,
              enable_graph=False, enable_prefix_cache=True, host_kv_blocks=4, enable_kvcache_store=True,
              kvcache_store_path=str(tmp_path))
    llm = LLM("tiny", **kw)
    eng = llm.engine
    g = torch.Generator().manual_seed(5)
    a = torch.randint(0, 32000, (100,), generator=g).tolist()
    others = [torch.randint(0, 32000, (120,), generator=g).tolist() for _ in range(4)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    first = llm.generate([a], sp)[0].outputs[0].token_ids
    for o in others:
        llm.generate([o], sp)
    st = eng.host_tier.stats()
    assert st["dropped"] >= 6 and st["store_saved"] >= 6, st
    chain = eng.rt.block_hash_chain(a, 16, 0)
    assert all(eng.host_tier.ext.contains(k) for k in chain[:6])
    assert eng.scheduler.block_manager(0).lookup(*chain[0]) < 0 and tuple(chain[0]) not in eng.host_tier.index
    again = llm.generate([a], sp)[0].outputs[0].token_ids
    assert again == first and eng.host_tier.stats()["store_loaded"] >= 6
    # a fresh engine with the same weights (the tiny preset is seeded) starts with the store already filled
    llm2 = LLM("tiny", **kw)
    q0 = llm2.engine.scheduler.block_stats(0).match_hits_blocks
    assert llm2.generate([a], sp)[0].outputs[0].token_ids == first
    assert llm2.engine.host_tier.stats()["store_loaded"] >= 6
    assert llm2.engine.scheduler.block_stats(0).match_hits_blocks - q0 >= 6
    # a different cache geometry never reads these files
    from xllm_b200.engine.host_tier import DirectoryKVStore
    other = DirectoryKVStore(str(tmp_path), "another-geometry")
    assert not other.contains(tuple(chain[0]))
    # capacity: the store trims its least recently used files
    small = DirectoryKVStore(str(tmp_path), "small", capacity_bytes=3000)
    for i in range(5):
        small.put((i, i), torch.full((1000,), i, dtype=torch.uint8))
    assert sum(small.contains((i, i)) for i in range(5)) == 3 and small.contains((4, 4))
