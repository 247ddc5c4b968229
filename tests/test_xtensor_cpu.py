"""The virtual-memory page pool on its host emulation: on-demand mapping, stable addresses across
sleep / wake-up, pages shared between two "models", exhaustion and trimming."""
import pytest
import torch

from xllm_b200.utils.xtensor import VmmPool


def test_map_on_demand_and_stable_addresses():
    pool = VmmPool(page_bytes=64 * 1024, max_pages=8, fake=True)
    pb = pool.page_bytes
    r = pool.range(6 * pb)
    assert r.mapped_bytes == 0 and pool.pages_in_use == 0
    r.ensure(2 * pb + 1)                               # three pages
    assert r.mapped_bytes == 3 * pb and pool.pages_in_use == 3
    t = r.tensor((3 * pb // 4,), torch.float32)
    t.copy_(torch.arange(t.numel(), dtype=torch.float32))
    addr = t.data_ptr()
    assert addr == r.ptr
    r.ensure(pb)                                       # already mapped: nothing changes
    assert pool.pages_in_use == 3 and float(t[-1]) == t.numel() - 1
    r.release_all()                                    # sleep
    assert r.mapped_bytes == 0 and pool.pages_in_use == 0 and pool.pages_free == 3
    r.ensure(3 * pb)                                   # wake up on recycled pages, same address
    assert pool.pages_created == 3 and r.tensor((4,), torch.float32).data_ptr() == addr


def test_two_models_share_the_pool():
    pool = VmmPool(page_bytes=64 * 1024, max_pages=4, fake=True)
    pb = pool.page_bytes
    a, b = pool.range(4 * pb), pool.range(4 * pb)
    a.ensure(4 * pb)
    with pytest.raises(RuntimeError):                  # model A holds every page
        b.ensure(pb)
    assert b.mapped_bytes == 0
    a.release_all()                                    # A sleeps, B wakes up on A's pages
    b.ensure(4 * pb)
    tb = b.tensor((pb,), torch.uint8, offset=3 * pb)
    tb.fill_(7)
    assert pool.pages_created == 4 and pool.pages_in_use == 4 and int(tb.sum()) == 7 * pb
    b.unmap_range(2 * pb, 2 * pb)                      # shrink B by two pages
    assert b.mapped_bytes == 2 * pb and pool.pages_free == 2
    assert pool.trim() == 2 and pool.pages_created == 2


def test_partial_ranges_round_to_pages():
    pool = VmmPool(page_bytes=64 * 1024, max_pages=8, fake=True)
    pb = pool.page_bytes
    r = pool.range(5 * pb)
    r.map_range(pb + 10, pb)                           # touches pages 1 and 2
    assert r.mapped_bytes == 2 * pb and r.x.is_mapped(pb) and not r.x.is_mapped(0)
    r.unmap_range(pb + 10, pb)                         # contains no whole page
    assert r.mapped_bytes == 2 * pb
    r.unmap_range(pb, 2 * pb)
    assert r.mapped_bytes == 0
    with pytest.raises(ValueError):
        r.tensor((6 * pb,), torch.uint8)


def test_engine_kv_cache_on_the_shared_page_pool_survives_sleep():
    """enable_xtensor: the KV cache lives on the device's page pool; sleep returns the pages (another
    engine can take them), wake-up maps pages again at the same address and generation repeats."""
    import torch
    from xllm_b200 import LLM, SamplingParams
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    from xllm_b200.utils.xtensor import shared_pool
    pool = shared_pool("cpu")
    kw = dict(model="tiny", device="cpu", dtype="float32", num_blocks=64, enable_graph=False, max_seqs_per_batch=4,
              max_tokens_per_batch=128, enable_xtensor=True)
    free0 = pool.pages_in_use
    a = LLMEngine(EngineConfig(**kw))
    used_a = pool.pages_in_use - free0
    assert used_a > 0 and a._kv_range is not None
    addr = a.runner.kv_tensor.data_ptr()
    llm = LLM.__new__(LLM)
    llm.engine, llm.tokenizer = a, None
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (20, 45)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    a.sleep(1)
    assert pool.pages_in_use == free0                      # every page of the cache went back
    b = LLMEngine(EngineConfig(**kw))                      # a second model takes pages of the same pool meanwhile
    assert pool.pages_in_use - free0 == used_a
    b.sleep(1)
    a.wake_up()
    assert a.runner.kv_tensor.data_ptr() == addr and pool.pages_in_use - free0 == used_a
    assert [o.outputs[0].token_ids for o in llm.generate(prompts, sp)] == want
