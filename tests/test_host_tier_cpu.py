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
